"""Each mechanism of Zokanex alone: the kernel or part against the plain function of the same name."""
import pytest
import torch

import plain_zokanex as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


def i32(values):
    return torch.tensor(values, dtype=torch.int32, device=DEV)


# ------------------------------------------------------------------ the heads' norm and the rotation of halves

@pytest.mark.parametrize("pad", [0, 3])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,dims,kv_heads,normed", [(40, 40, 2, (True, True)), (32, 16, 1, (True, True)), (64, 24, 0, (True, False)),
                                                      (20, 10, 3, (False, True)), (128, 0, 2, (True, True)), (12, 12, 0, (False, False))])
def test_heads_are_normed_and_rotated_in_one_pass(dim, dims, kv_heads, normed, dtype, pad):
    from damendaemon_b200 import kernels
    H, G, T, eps = 3, kv_heads, 11, 1e-5
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 1000, 2047, 2048, 5000, 7], dtype=torch.int32)
    buf = rnd(T, (H + G) * dim + pad, seed=4, scale=3.0).to(dtype)
    wq, wk = 1.0 + rnd(dim, seed=5, scale=0.2), 1.0 + rnd(dim, seed=6, scale=0.2)
    q64 = buf[:, :H * dim].double().view(T, H, dim)
    k64 = buf[:, H * dim:(H + G) * dim].double().view(T, G, dim)
    want_q = plain.rms_norm(q64, wq.double(), eps) if normed[0] else q64
    want_k = plain.rms_norm(k64, wk.double(), eps) if normed[1] else k64
    if dims:
        want_q, want_k = (plain.rotate_halves(x, positions, dims, 5000.0) for x in (want_q, want_k))
    dev = buf.to(DEV)
    q, k = dev[:, :H * dim], (dev[:, H * dim:(H + G) * dim] if G else None)
    freqs = None
    if dims:
        freqs = (5000.0 ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float().to(DEV)
    kernels.head_norm_rotary(q, k, positions.to(DEV), wq.to(DEV) if normed[0] else None, wk.to(DEV) if normed[1] and G else None,
                             eps, H, G, dim, freqs=freqs, interleaved=False)
    tol = 1e-3 if dtype == torch.float32 else 0.05           # an angle of thousands of radians in float32
    assert (dev[:, :H * dim].cpu().double().view(T, H, dim) - want_q).abs().max() < tol
    if G:
        assert (dev[:, H * dim:(H + G) * dim].cpu().double().view(T, G, dim) - want_k).abs().max() < tol
    if pad:
        assert torch.equal(dev[:, (H + G) * dim:].cpu(), buf[:, (H + G) * dim:])       # what lies behind the heads is untouched


# ------------------------------------------------------------------ retention

def new_state(n_slots, H, dk, dv, fill=0.0):
    from damendaemon_b200 import kernels
    return torch.full((n_slots, *kernels.retention_state_shape(H, dk, dv)), fill, device=DEV)


def run_retention(q, k, v, lengths, slots, decay, key_scale, state, dims, base, dtype, interleaved=False):
    """One launch over entries of the given lengths (rows side by side) whose requests sit in the given slots and have
    state['pos'][slot] tokens behind them already."""
    from damendaemon_b200 import kernels
    starts = [0]
    for n in lengths:
        starts.append(starts[-1] + n)
    positions = torch.cat([torch.arange(state["pos"][s], state["pos"][s] + n) for s, n in zip(slots, lengths)]).to(torch.int32)
    buf = torch.cat([q, k, v], dim=1).to(dtype).to(DEV)
    qd, kd, vd = buf.split([q.shape[1], k.shape[1], v.shape[1]], dim=1)
    freqs = None if not dims else (base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).float().to(DEV)
    out = kernels.retention(qd, kd, vd, positions.to(DEV), i32(starts), i32(slots), torch.tensor(decay, dtype=torch.float32, device=DEV),
                            key_scale, state["S"], q.shape[1] // len(decay), v.shape[1] // len(decay), freqs=freqs, interleaved=interleaved)
    assert kernels.read_error_flag(DEV) == 0
    for s, n in zip(slots, lengths):
        state["pos"][s] += n
    return out.cpu().double(), starts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dk,dv,dims,decay", [(2, 16, 24, 8, [0.9, 0.97]), (3, 8, 8, 0, [1.0, 0.5, 0.0]), (4, 64, 64, 32, [0.99, 0.995, 0.999, 0.9]),
                                                (2, 40, 36, 20, [0.98, 0.8]), (2, 128, 64, 128, [0.97, 0.999]), (1, 256, 40, 64, [0.95]),
                                                (1, 1, 1, 0, [0.5])])
def test_retention_in_portions_against_the_recurrence(H, dk, dv, dims, decay, dtype):
    """Four requests of unequal length in shuffled slots: a first step of portions (1, 5, 17 and 40 tokens), then more
    portions down to two tokens and single tokens, one request left out of a step; every output equals the plain
    recurrence over the whole sequence, whose state the kernel must therefore have carried."""
    n_slots, total = 6, [60, 9, 40, 58]
    slots = [4, 0, 5, 2]
    seqs = [(rnd(n, H * dk, seed=10 + i), rnd(n, H * dk, seed=20 + i), rnd(n, H * dv, seed=30 + i)) for i, n in enumerate(total)]
    scale = dk ** -0.5
    want = []
    for (q, k, v), n in zip(seqs, total):
        q64, k64, v64 = (t.to(dtype).double().view(n, H, -1) for t in (q, k, v))
        if dims:
            pos = torch.arange(n)
            q64, k64 = plain.rotate_halves(q64, pos, dims, 300.0), plain.rotate_halves(k64, pos, dims, 300.0)
        want.append(plain.retention_recurrence(q64, k64 * scale, v64, torch.tensor(decay, dtype=torch.float64))[0].reshape(n, H * dv))
    state = {"S": new_state(n_slots, H, dk, dv, float("nan")), "pos": [0] * n_slots}
    for s in slots:
        state["S"][s].zero_()                                  # what taking a slot does
    at = [0] * 4
    steps = [[1, 5, 17, 40], [2, 1, 16, 1], [33, 1, 0, 2], [1, 2, 7, 1], [23, 0, 0, 14]]
    tol = 2e-5 if dtype == torch.float32 else 2e-4              # float32 inside, whatever the storage type of q, k, v
    for lengths in steps:
        live = [i for i, n in enumerate(lengths) if n]
        q, k, v = (torch.cat([seqs[i][j][at[i]:at[i] + lengths[i]] for i in live]) for j in range(3))
        out, starts = run_retention(q, k, v, [lengths[i] for i in live], [slots[i] for i in live], decay, scale, state, dims, 300.0, dtype)
        for j, i in enumerate(live):
            got = out[starts[j]:starts[j + 1]]
            ref = want[i][at[i]:at[i] + lengths[i]]
            assert (got - ref).abs().max() < tol * max(1.0, ref.abs().max().item()), (i, at[i], lengths[i])
            at[i] += lengths[i]
    assert at == total
    assert torch.isnan(state["S"][1]).all() and torch.isnan(state["S"][3]).all()      # other slots are never touched


def test_a_slot_taken_again_starts_from_zero_and_a_prompt_equals_its_tokens_one_by_one():
    H, dk, dv, n = 2, 32, 48, 70
    q, k, v = rnd(n, H * dk, seed=1), rnd(n, H * dk, seed=2), rnd(n, H * dv, seed=3)
    state = {"S": new_state(2, H, dk, dv), "pos": [0, 0]}
    whole, _ = run_retention(q, k, v, [n], [1], [0.9, 0.99], 0.2, state, 16, 100.0, torch.float32)
    kept = state["S"][1].clone()
    # the same slot again, as a new request: zeroed, then token by token
    state["S"][1].zero_()
    state["pos"][1] = 0
    single = torch.cat([run_retention(q[t:t + 1], k[t:t + 1], v[t:t + 1], [1], [1], [0.9, 0.99], 0.2, state, 16, 100.0, torch.float32)[0]
                        for t in range(n)])
    assert torch.equal(whole, single)          # one arithmetic, one order: a prompt's cut changes no bit
    assert torch.equal(kept, state["S"][1])


@pytest.mark.parametrize("decay", [1.0, 0.999])
def test_a_marked_token_far_back_reaches_the_read_out_through_the_state(decay):
    """Among 700 tokens one, near the start, has a key that the last query alone is aligned with; every other key is
    orthogonal to that query: the last output is that token's value times decay^distance, in one prompt step and when
    the last 30 tokens come one by one."""
    H, dk, dv, n, far = 1, 16, 8, 700, 3
    q, k, v = rnd(n, dk, seed=4, scale=0.5), rnd(n, dk, seed=5, scale=0.5), rnd(n, dv, seed=6)
    k[:, 0] = 0.0
    q[:, 0] = 0.0
    k[far, 0], q[n - 1, :] = 7.0, 0.0
    q[n - 1, 0] = 3.0
    want = v[far].double() * 21.0 * decay ** (n - 1 - far)
    state = {"S": new_state(1, H, dk, dv), "pos": [0]}
    whole, _ = run_retention(q, k, v, [n], [0], [decay], 1.0, state, 0, 1.0, torch.float32)
    assert (whole[n - 1] - want).abs().max() < 2e-4 * want.abs().max()
    state = {"S": new_state(1, H, dk, dv), "pos": [0]}
    run_retention(q[:n - 30], k[:n - 30], v[:n - 30], [n - 30], [0], [decay], 1.0, state, 0, 1.0, torch.float32)
    for t in range(n - 30, n):
        last, _ = run_retention(q[t:t + 1], k[t:t + 1], v[t:t + 1], [1], [0], [decay], 1.0, state, 0, 1.0, torch.float32)
    assert (last[0] - want).abs().max() < 2e-4 * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,dv", [(2, 24), (4, 64), (3, 36), (1, 1)])
def test_the_read_out_is_divided_by_its_root_mean_square_and_gated(H, dv, dtype):
    from damendaemon_b200 import kernels
    T, eps = 13, 1e-5
    o, gate = rnd(T, H * dv, seed=7, scale=4.0), rnd(T, H * dv + 5, seed=8, scale=2.0).to(dtype)
    g = gate[:, :H * dv].double()
    want = (plain.rms_norm(o.double().view(T, H, dv), None, eps).reshape(T, H * dv) * plain.silu(g))
    got = kernels.retention_finish(o.to(DEV), gate.to(DEV)[:, :H * dv], H, eps, dtype).cpu().double()
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.05)


# ------------------------------------------------------------------ feed-forwards

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("form", ["silu", "gelu_tanh"])
def test_the_gated_units_forms(form, dtype):
    from damendaemon_b200 import kernels
    rows, inner = 37, 52
    gate_up, by = rnd(rows, 2 * inner, seed=9, scale=3.0).to(dtype), rnd(rows, seed=10).abs()
    act = plain.silu if form == "silu" else plain.gelu_tanh
    want = act(gate_up[:, :inner].double()) * gate_up[:, inner:].double()
    got = kernels.gated_unit(gate_up.to(DEV), 0.0, 1.0, form=form).cpu().double()
    tol = 1e-6 if dtype == torch.float32 else 0.01            # of a value's size: bfloat16 keeps eight bits of it
    assert ((got - want).abs() / want.abs().clamp(min=1.0)).max() < tol
    got = kernels.gated_unit(gate_up.to(DEV), 0.0, 1.0, form=form, row_scale=by.to(DEV)).cpu().double()
    want = want * by.double()[:, None]
    assert ((got - want).abs() / want.abs().clamp(min=1.0)).max() < tol


def part_context(tokens, runtime, ids=None):
    from damendaemon_b200.engine.context import StepContext
    return StepContext(n_tokens=tokens, n_entries=1, n_wanted=0, token_ids=ids, positions=None, token_entry=None, want_rows=None,
                       entry_slot=None, entry_start=None, entry_pos0=None, block_tables={}, runtime=runtime)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,inner,tokens", [(64, 96, 1), (100, 52, 37), (256, 512, 200)])
def test_the_dense_gated_feed_forward(width, inner, tokens, dtype):
    from damendaemon_b200.parts import GatedFeedForwardSpec, GatedUnitSpec, Runtime
    from damendaemon_b200.parts.feed_forward import GatedFeedForward
    w = {"gate": rnd(inner, width, seed=11, scale=width ** -0.5), "up": rnd(inner, width, seed=12, scale=width ** -0.5),
         "down": rnd(width, inner, seed=13, scale=inner ** -0.5)}
    y, stream = rnd(tokens, width, seed=14), rnd(tokens, width, seed=15)
    rounded = {k: t.to(dtype).double() for k, t in w.items()}
    want = stream.double() + plain.gated_ff(y.to(dtype).double(), rounded, plain.gelu_tanh)
    runtime = Runtime(dtype=dtype, device=torch.device(DEV))
    spec = GatedFeedForwardSpec("gated", width, GatedUnitSpec(inner, 0.0, "gate", "up", "down", alpha=1.0, activation="gelu_tanh"))
    weights = {"gate+up": torch.cat([w["gate"], w["up"]]).to(dtype).to(DEV), "down": w["down"].to(dtype).to(DEV)}
    got = GatedFeedForward(spec, weights, runtime).forward(y.to(dtype).to(DEV), stream.clone().to(DEV), part_context(tokens, runtime))
    assert (got.cpu().double() - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.05)


@pytest.mark.parametrize("dtype,width", [(torch.float32, 64), (torch.bfloat16, 256), (torch.float32, 99), (torch.bfloat16, 100)])
@pytest.mark.parametrize("experts,top,groups,keep", [(8, 2, 4, 2), (16, 3, 2, 1), (6, 2, 3, 1), (5, 1, 1, 1), (6, 2, 6, 2), (3, 3, 1, 1),
                                                     (64, 6, 8, 3), (12, 4, 4, 4)])
def test_the_router_chooses_within_the_worthiest_groups(experts, top, groups, keep, dtype, width):
    from damendaemon_b200 import kernels
    tokens = 300
    y = rnd(tokens, width + (3 if width % 8 else 0), seed=experts + top, scale=1.0).to(dtype)[:, :width]      # odd widths: a padded row stride too
    router = rnd(experts + 1, width, seed=experts, scale=2.0 * width ** -0.5).to(dtype)
    logits = y.double() @ router.double().T
    scores = torch.sigmoid(logits[:, :experts])
    want = plain.choose_experts(scores, top, groups, keep)
    chosen, weight, shared = kernels.route_by_score(y.to(DEV), router.to(DEV), experts, top, groups, keep, 2.5, shared_gate=True)
    assert torch.equal(chosen.cpu().long(), want)
    assert (weight.cpu().double() - 2.5 * scores.gather(1, want)).abs().max() < 2e-6
    assert (shared.cpu().double() - torch.sigmoid(logits[:, experts])).abs().max() < 2e-6
    # one group holds every expert: the plain top scores; and no shared unit
    chosen, _, none = kernels.route_by_score(y.to(DEV), router[:experts].to(DEV), experts, top, 1, 1, 1.0)
    assert none is None and torch.equal(chosen.cpu().long(), scores.topk(top, dim=-1).indices)


def test_a_group_wins_by_its_two_best_and_loses_its_best_expert_with_it():
    """The largest single score lies in a group whose second score is small: with one group kept, that expert is not chosen."""
    from damendaemon_b200 import kernels
    router = torch.zeros(6, 8)
    router[:, 0] = torch.tensor([4.0, -6.0, -6.0, 1.0, 1.5, -6.0])
    y = torch.zeros(1, 8)
    y[0, 0] = 1.0
    chosen, weight, _ = kernels.route_by_score(y.to(DEV), router.to(DEV), 6, 2, 2, 1, 1.0)
    assert chosen.cpu().tolist() == [[4, 3]]
    assert weight.cpu()[0, 0].item() == pytest.approx(torch.sigmoid(torch.tensor(1.5)).item(), abs=1e-6)
    chosen, _, _ = kernels.route_by_score(y.to(DEV), router.to(DEV), 6, 2, 2, 2, 1.0)
    assert chosen.cpu().tolist() == [[0, 4]]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,groups,keep,shared,tokens", [(8, 2, 4, 2, 40, 1), (8, 2, 4, 2, 40, 37), (6, 2, 3, 1, 12, 200),
                                                                   (5, 1, 1, 1, None, 60), (3, 3, 1, 1, 16, 5), (16, 3, 2, 1, 24, 70)])
def test_experts_chosen_by_score(experts, top, groups, keep, shared, tokens, dtype):
    from damendaemon_b200.parts import GatedUnitSpec, Runtime, ScoreRoutedExpertsSpec
    from damendaemon_b200.parts.feed_forward import ScoreRoutedExperts
    width, inner, scale = 64, 24, 1.75
    w = {}
    for e in list(range(experts)) + (["s"] if shared else []):
        p = "shared." if e == "s" else f"e{e}."
        size = shared if e == "s" else inner
        w[p + "gate"], w[p + "up"] = rnd(size, width, seed=20 + len(w), scale=0.3), rnd(size, width, seed=21 + len(w), scale=0.3)
        w[p + "down"] = rnd(width, size, seed=22 + len(w), scale=0.3)
    w["router"] = rnd(experts, width, seed=3, scale=0.4)
    if shared:
        w["shared.sg"] = rnd(1, width, seed=4, scale=0.3)
    y, stream = rnd(tokens, width, seed=30), rnd(tokens, width, seed=31)
    rounded = {k: t.to(dtype).double() for k, t in w.items()}
    c = {"router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}, "shared": {"ff": shared} if shared else None}
    want = stream.double() + plain.routed_experts(y.to(dtype).double(), rounded, c)
    unit = lambda p, size: GatedUnitSpec(size, 0.0, p + "gate", p + "up", p + "down", alpha=1.0, activation="silu")
    spec = ScoreRoutedExpertsSpec("experts_by_score", width, top, "router", tuple(unit(f"e{e}.", inner) for e in range(experts)),
                                  groups=groups, keep_groups=keep, weight_scale=scale, shared=unit("shared.", shared) if shared else None,
                                  shared_gate="shared.sg" if shared else None)
    runtime = Runtime(dtype=dtype, device=torch.device(DEV))
    weights = {k: t.to(dtype).to(DEV) for k, t in w.items()}
    if shared:
        weights["router+shared.sg"] = torch.cat([weights.pop("router"), weights.pop("shared.sg")])
    part = ScoreRoutedExperts(spec, weights, runtime)
    got = part.forward(y.to(dtype).to(DEV), stream.clone().to(DEV), part_context(tokens, runtime)).cpu().double()
    assert (got - want).abs().max() < (3e-6 if dtype == torch.float32 else 0.01) * max(1.0, want.abs().max().item())


# ------------------------------------------------------------------ windows

def cache_for(k, v, kv_heads, dim, vdim, page, dtype, seed):
    """The keys and values of one request in shuffled pages of a poisoned pool."""
    from damendaemon_b200 import kernels
    T = k.shape[0]
    n_pages = -(-T // page) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed))[: -(-T // page)].to(torch.int32)
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, :order.numel()] = order
    buf = torch.cat([k, v], dim=1).to(dtype).to(DEV)
    kd, vd = buf.split([kv_heads * dim, kv_heads * vdim], dim=1)
    if dim == vdim:
        cache = torch.full((n_pages, 2, kv_heads, page, dim), float("nan"), dtype=dtype, device=DEV)
    else:
        cache = torch.full((n_pages, kv_heads * page * (dim + vdim)), float("nan"), dtype=dtype, device=DEV)
    kernels.kv_store(kd, vd, torch.zeros(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV),
                     table.to(DEV), cache, kv_heads=kv_heads, head_dim=dim, v_dim=vdim)
    return cache, table.to(DEV)


def attend(q, cache, table, rows, heads, kv_heads, vdim, scale, window, splits=1):
    """The queries of the given positions, as one step (a portion if they are consecutive, else single tokens of one
    request run one after the other)."""
    from damendaemon_b200 import kernels
    out = {}
    runs = [rows] if rows == list(range(rows[0], rows[0] + len(rows))) else [[r] for r in rows]
    for run in runs:
        qd = q[run[0]:run[0] + len(run)].contiguous().to(cache.dtype).to(DEV)
        got = kernels.attention_rows(qd, cache, torch.zeros(len(run), dtype=torch.int32, device=DEV), i32(run), table, heads, scale,
                                     window, n_splits=splits if len(run) == 1 else 1, kv_heads=kv_heads, v_dim=vdim).cpu().double()
        out.update({r: got[i] for i, r in enumerate(run)})
    assert kernels.read_error_flag(DEV) == 0
    return out


@pytest.mark.parametrize("window,page", [(24, 16), (33, 16), (7, 8), (100, 16), (16, 16), (1, 8)])
def test_a_key_just_inside_and_just_outside_the_window(window, page):
    """A query looks for three marked keys: the oldest one its window still holds, the one just before that, and the
    very first key of the sequence. Only the first of the three may be found: the output is that key's value, whether the
    query comes in a portion of a prompt or alone, with its keys cut into pieces or not; and the first tokens of the
    sequence, whose window reaches before the start, see what there is."""
    heads, kv_heads, dim, vdim, T = 4, 2, 16, 8, 3 * max(window, 8) + 5
    q, k = rnd(T, heads * dim, seed=9, scale=0.1), rnd(T, kv_heads * dim, seed=10, scale=0.1)
    v = rnd(T, kv_heads * vdim, seed=11)
    last = T - 1
    oldest = last - window + 1
    for h in range(kv_heads):
        k[oldest, h * dim + 0] = 40.0
        if oldest > 0:
            k[oldest - 1, h * dim + 1] = 45.0            # a stronger mark, just outside
        k[0, h * dim + 2] = 50.0                         # the strongest, far outside
    for h in range(heads):
        q[last, h * dim:h * dim + 3] = 1.0
        q[min(window, T) - 1, h * dim + 2] = 1.0         # the last query whose window still holds key 0
        q[min(window, T - 1), h * dim + 2] = 1.0         # the first one whose window does not
    cache, table = cache_for(k, v, kv_heads, dim, vdim, page, torch.float32, seed=1)
    value = lambda p: torch.cat([v[p, (h * kv_heads // heads) * vdim:(h * kv_heads // heads + 1) * vdim] for h in range(heads)]).double()
    exact = plain.grouped_softmax_attention(q.double().view(T, heads, dim), k.double().view(T, kv_heads, dim),
                                            v.double().view(T, kv_heads, vdim), 1.0, plain.window_visible(T, window)).reshape(T, -1)
    portion = attend(q, cache, table, list(range(T - 9, T)), heads, kv_heads, vdim, 1.0, window)
    single = attend(q, cache, table, [last, window - 1, min(window, T - 1), 0], heads, kv_heads, vdim, 1.0, window, splits=3)
    for got in (portion[last], single[last]):
        assert (got - value(oldest)).abs().max() < 1e-3
    assert (single[window - 1] - value(0)).abs().max() < 1e-3
    assert (single[0] - value(0)).abs().max() < 1e-6
    if window > 1:
        assert (single[min(window, T - 1)] - value(0)).abs().max() > 0.1          # key 0 has just left the window
    for rows in (portion, single):
        for p, row in rows.items():
            assert (row - exact[p]).abs().max() < 1e-4, p


@pytest.mark.parametrize("kernel", ["tcgen05", "mma", "decode"])
def test_the_tensor_core_kernels_take_queries_alone_and_respect_the_window(kernel):
    """Heads of 64 in bfloat16, the keys in the cache already (another layer wrote them): prompt portions through both
    prompt kernels and single tokens through the decode kernel, with no keys or values handed in, against the plain
    attention under the same window; the marked key just outside the window leaves no trace."""
    from damendaemon_b200 import kernels
    heads, kv_heads, dim, T, window, page = 4, 4, 64, 300, 100, 16
    if kernel == "tcgen05" and not kernels.attention_prefill_tcgen05_supported(heads, kv_heads, dim, page, torch.bfloat16):
        pytest.skip("sizes the tcgen05 prompt kernel does not take")
    q, k, v = rnd(T, heads * dim, seed=12, scale=0.3), rnd(T, kv_heads * dim, seed=13, scale=0.3), rnd(T, kv_heads * dim, seed=14)
    last = T - 1
    for h in range(heads):
        k[last - window + 1, h * dim] = 400.0
        k[last - window, h * dim + 1] = 420.0
        q[last, h * dim:h * dim + 2] = 1.0
    cache, table = cache_for(k, v, kv_heads, dim, dim, page, torch.bfloat16, seed=2)
    r = lambda t: t.bfloat16().double()
    exact = plain.grouped_softmax_attention(r(q).view(T, heads, dim), r(k).view(T, kv_heads, dim), r(v).view(T, kv_heads, dim),
                                            0.125, plain.window_visible(T, window)).reshape(T, -1)
    first = 150
    qd = q[first:].bfloat16().to(DEV)
    if kernel == "decode":
        rows = [last, last - 1, first]
        got = {}
        for p in rows:
            got[p] = kernels.attention_decode(q[p:p + 1].bfloat16().to(DEV), cache, None, i32([p]), table, heads, 0.125, window,
                                              n_splits=2)[0].cpu().double()
    else:
        out = kernels.attention_prefill(qd, cache, i32([0, T - first]), i32([first]), table, heads, 0.125, window, kernel=kernel).cpu().double()
        got = {first + i: out[i] for i in range(T - first)}
    assert kernels.read_error_flag(DEV) == 0
    for p, row in got.items():
        assert (row - exact[p]).abs().max() < 0.03, p
    assert (got[last] - r(v)[last - window + 1]).abs().max() < 0.03

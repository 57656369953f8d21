"""Each mechanism of Bonatar alone: the kernel against the plain function of the same name."""
import math

import pytest
import torch

import plain_bonatar as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g) * scale


@pytest.mark.parametrize("width", [48, 328, 2052, 4100])
def test_rms_norm_with_a_weight_stored_around_zero(width):
    from damendaemon_b200 import kernels
    x, w = rnd(9, width, seed=1, scale=7.0), rnd(width, seed=2, scale=0.3)
    want = plain.rms_norm_offset(x.double(), w.double(), 1e-5)
    got = kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, torch.float32, offset=1.0).cpu()
    assert (got - want).abs().max() < 1e-5
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    got = kernels.rmsnorm(x.to(DEV), w.to(DEV), 1e-5, torch.bfloat16, row_index=rows.to(DEV), offset=1.0).cpu().double()
    assert (got - want[rows.long()]).abs().max() < 0.03
    # offset 0: the weight is the factor itself
    got = kernels.rmsnorm(x.to(DEV), (1.0 + w).to(DEV), 1e-5, torch.float32).cpu()
    assert (got - want).abs().max() < 1e-5


def test_embedding_scale():
    from damendaemon_b200 import kernels
    table = rnd(50, 24, seed=3)
    ids = torch.tensor([4, 49, 0, 4], dtype=torch.int32)
    got = kernels.embed(ids.to(DEV), torch.zeros(4, dtype=torch.int32, device=DEV), table.to(DEV), scale=5.25).cpu()
    assert torch.equal(got, plain.embed(ids.long(), table, 5.25))


@pytest.mark.parametrize("pad", [5, 6])       # odd row stride: element by element; even: a pair is one word
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,dims,scaling", [(40, 40, None), (32, 16, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}),
                                              (64, 24, {"factor": 3.0, "original": 1024, "fast": 16.0, "slow": 2.0})])
def test_rotary_pairs_of_neighbours_on_part_of_a_head(dim, dims, scaling, dtype, pad):
    from damendaemon_b200 import kernels
    from damendaemon_b200.parts.positions import rotary_frequencies
    from damendaemon_b200.parts.spec import LongContextBlend, RotarySpec
    H, G, T = 3, 2, 11
    positions = torch.tensor([0, 1, 2, 63, 64, 65, 1000, 2047, 2048, 5000, 7], dtype=torch.int32)
    buf = rnd(T, (H + G) * dim + pad, seed=4).to(dtype)
    want_f, want_m = plain.rotary_frequencies(dims, 5000.0, scaling)
    spec = RotarySpec("rotary", dim, dims, 5000.0, True, None if scaling is None else LongContextBlend(**scaling))
    freqs, magnitude = rotary_frequencies(spec)
    assert torch.allclose(freqs, want_f, rtol=1e-12) and magnitude == pytest.approx(want_m)
    if scaling is not None:
        plain_f = plain.rotary_frequencies(dims, 5000.0)[0]
        assert (freqs[0] == plain_f[0]) and freqs[-1] == pytest.approx(plain_f[-1] / scaling["factor"])   # both ends of the blend
    dev = buf.to(DEV)
    q, k = dev[:, :H * dim], dev[:, H * dim:(H + G) * dim]
    kernels.rotary(q, k, positions.to(DEV), freqs.float().to(DEV), magnitude, H, G, dim)
    want_q = plain.rotate_pairs(buf[:, :H * dim].double().view(T, H, dim), positions, want_f, want_m).view(T, -1)
    want_k = plain.rotate_pairs(buf[:, H * dim:(H + G) * dim].double().view(T, G, dim), positions, want_f, want_m).view(T, -1)
    tol = 2e-3 if dtype == torch.float32 else 0.05     # float32 angles of thousands of radians carry 1e-4 of error
    assert (q.cpu().double() - want_q).abs().max() < tol and (k.cpu().double() - want_k).abs().max() < tol
    assert torch.equal(dev[:, (H + G) * dim:].cpu(), buf[:, (H + G) * dim:])        # what follows the keys is untouched
    if dims < dim:
        assert torch.equal(q.cpu().view(T, H, dim)[..., dims:], buf[:, :H * dim].view(T, H, dim)[..., dims:])
    small = positions < 100
    assert (q.cpu().double() - want_q)[small].abs().max() < (1e-5 if dtype == torch.float32 else 0.05)


def attend_alone(q, k, v, gate, heads, kv_heads, dim, vdim, scale, chunk, dtype, page=8, splits=1, window=None):
    """One request whose T tokens are written to shuffled pages and attended in one step by the general kernel."""
    from damendaemon_b200 import kernels
    T = q.shape[0]
    n_pages = -(-T // page) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(1))[: -(-T // page)].to(torch.int32)
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, :order.numel()] = order
    buf = torch.cat([q, k, v, gate], dim=1).to(dtype).to(DEV)
    widths = [heads * dim, kv_heads * dim, kv_heads * vdim, heads]
    qd, kd, vd, gd = buf.split(widths, dim=1)
    if dim == vdim:
        cache = torch.full((n_pages, 2, kv_heads, page, dim), float("nan"), dtype=dtype, device=DEV)
    else:
        cache = torch.full((n_pages, kv_heads * page * (dim + vdim)), float("nan"), dtype=dtype, device=DEV)
    entry = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    kernels.kv_store(kd, vd, entry, pos, table.to(DEV), cache, kv_heads=kv_heads, head_dim=dim, v_dim=vdim)
    out = kernels.attention_rows(qd, cache, entry, pos, table.to(DEV), heads, scale, window, n_splits=splits, chunk=chunk,
                                 gate=gd, kv_heads=kv_heads, v_dim=vdim)
    assert kernels.read_error_flag(DEV) == 0
    return out.cpu().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,chunk,splits", [(4, 2, 40, 40, 56, 1), (4, 2, 32, 16, 24, 3), (3, 3, 16, 40, 7, 1),
                                                                  (2, 1, 64, 64, None, 4), (6, 2, 12, 20, 10, 2)])
def test_chunked_gated_attention_with_grouped_heads(heads, kv_heads, dim, vdim, chunk, splits, dtype):
    T = 150
    q, k = rnd(T, heads * dim, seed=5, scale=1.5), rnd(T, kv_heads * dim, seed=6, scale=1.5)
    v, gate = rnd(T, kv_heads * vdim, seed=7), rnd(T, heads, seed=8, scale=2.0)
    rounded = [t.to(dtype).double() for t in (q, k, v, gate)]
    want = plain.grouped_attention(rounded[0].view(T, heads, dim), rounded[1].view(T, kv_heads, dim),
                                   rounded[2].view(T, kv_heads, vdim), 0.3, plain.visible(T, chunk))
    want = (want * torch.sigmoid(rounded[3])[:, :, None]).reshape(T, heads * vdim)
    got = attend_alone(q, k, v, gate, heads, kv_heads, dim, vdim, 0.3, chunk, dtype, splits=splits)
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.02)


@pytest.mark.parametrize("chunk,page", [(48, 16), (24, 16), (7, 8), (100, 16)])
def test_a_key_just_inside_and_just_outside_a_chunk(chunk, page):
    """One key per probe is made to stand out (a large common component with the probing query): the output is that
    key's value when the key is in the query's chunk, and shows no trace of it when it is the last key of the chunk before."""
    heads, kv_heads, dim, vdim, T = 2, 1, 16, 8, 3 * chunk + 5
    q, k = rnd(T, heads * dim, seed=9, scale=0.1), rnd(T, kv_heads * dim, seed=10, scale=0.1)
    v, gate = rnd(T, kv_heads * vdim, seed=11), torch.full((T, heads), 30.0)      # sigmoid(30) = 1
    first, last = 2 * chunk, 3 * chunk - 1                    # first and last position of the third chunk
    k[first, 0] = k[first - 1, 1] = 40.0                      # dimension 0 marks the chunk's first key, dimension 1 the key before it
    k[0, 2] = 40.0                                            # dimension 2 marks the very first key of the sequence
    for h in range(heads):
        q[last, h * dim + 0] = q[last, h * dim + 1] = q[last, h * dim + 2] = 40.0     # sees `first` only
        q[first, h * dim + 1] = q[first, h * dim + 2] = 40.0                           # first of its chunk: sees itself only
        q[first - 1, h * dim + 1] = 40.0                                               # last of the chunk before: sees itself
    got = attend_alone(q, k, v, gate, heads, kv_heads, dim, vdim, 1.0, chunk, torch.float32, page=page)
    value = lambda p: v[p].double().repeat(heads)
    assert (got[last] - value(first)).abs().max() < 1e-4
    assert (got[first] - value(first)).abs().max() < 1e-4
    assert (got[first - 1] - value(first - 1)).abs().max() < 1e-4
    # and the first tokens of the sequence: position 0 sees itself, the last of the first chunk finds key 0 by its mark
    assert (got[0] - value(0)).abs().max() < 1e-4
    q2 = q.clone()
    for h in range(heads):
        q2[chunk - 1, h * dim + 2] = 40.0
        q2[chunk, h * dim + 2] = 40.0          # the next chunk's first query looks for key 0 and must not find it
    got2 = attend_alone(q2, k, v, gate, heads, kv_heads, dim, vdim, 1.0, chunk, torch.float32, page=page)
    assert (got2[chunk - 1] - value(0)).abs().max() < 1e-4
    assert (got2[chunk] - value(chunk)).abs().max() < 1e-4


def decode_alone(q, k, v, gate, heads, kv_heads, dim, vdim, scale, chunk, positions, page=8, splits=3):
    """All T tokens' keys and values are in shuffled pages; the queries at ``positions`` are attended one by one, each as a
    step of a single token with its keys cut into splits (what a decode step does)."""
    from damendaemon_b200 import kernels
    T = q.shape[0]
    n_pages = -(-T // page) + 2
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(2))[: -(-T // page)].to(torch.int32)
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, :order.numel()] = order
    buf = torch.cat([q, k, v, gate], dim=1).to(DEV)
    qd, kd, vd, gd = buf.split([heads * dim, kv_heads * dim, kv_heads * vdim, heads], dim=1)
    cache = torch.full((n_pages, kv_heads * page * (dim + vdim)), float("nan"), device=DEV) if dim != vdim else \
        torch.full((n_pages, 2, kv_heads, page, dim), float("nan"), device=DEV)
    entry = torch.zeros(T, dtype=torch.int32, device=DEV)
    kernels.kv_store(kd, vd, entry, torch.arange(T, dtype=torch.int32, device=DEV), table.to(DEV), cache, kv_heads=kv_heads,
                     head_dim=dim, v_dim=vdim)
    out = {}
    for p in positions:
        pos = torch.tensor([p], dtype=torch.int32, device=DEV)
        out[p] = kernels.attention_rows(qd[p:p + 1], cache, entry[:1], pos, table.to(DEV), heads, scale, None, n_splits=splits,
                                        chunk=chunk, gate=gd[p:p + 1], kv_heads=kv_heads, v_dim=vdim)[0].cpu().double()
    assert kernels.read_error_flag(DEV) == 0
    return out


@pytest.mark.parametrize("chunk", [None, 48, 100])
def test_a_marked_key_far_back_in_a_prompt_and_in_decoding(chunk):
    """Among 600 keys one, near the start, carries a mark that the last query looks for: without chunks the output is
    that key's value, in a prompt step and in a single-token step alike; with chunks the far key is not seen, and a key
    marked at the start of the last chunk is, while the one just before that start is not."""
    heads, kv_heads, dim, vdim, T = 2, 2, 16, 24, 600
    q, k = rnd(T, heads * dim, seed=40, scale=0.1), rnd(T, kv_heads * dim, seed=41, scale=0.1)
    v, gate = rnd(T, kv_heads * vdim, seed=42), torch.full((T, heads), 30.0)
    far, last = 3, T - 1
    start = 0 if chunk is None else last - last % chunk          # the first key the last query sees
    for h in range(kv_heads):
        k[far, h * dim + 0] = 50.0                               # dimension 0: the far key
        if chunk is not None:
            k[start, h * dim + 1] = 40.0                         # dimension 1: the first key of the last chunk (weaker than the far one)
            k[start - 1, h * dim + 2] = 45.0                     # dimension 2: the key just before it
    for h in range(heads):
        q[last, h * dim + 0] = q[last, h * dim + 1] = q[last, h * dim + 2] = 1.0
    seen = far if chunk is None else start
    want = torch.cat([v[seen, (h * kv_heads // heads) * vdim:(h * kv_heads // heads + 1) * vdim] for h in range(heads)]).double()
    whole = attend_alone(q, k, v, gate, heads, kv_heads, dim, vdim, 1.0, chunk, torch.float32, page=16, splits=1)
    assert (whole[last] - want).abs().max() < 1e-3
    single = decode_alone(q, k, v, gate, heads, kv_heads, dim, vdim, 1.0, chunk, [last, start, max(start - 1, 0)], page=16)
    assert (single[last] - want).abs().max() < 1e-3
    exact = plain.grouped_attention(q.double().view(T, heads, dim), k.double().view(T, kv_heads, dim), v.double().view(T, kv_heads, vdim),
                                    1.0, plain.visible(T, chunk)).reshape(T, -1)
    for p, row in single.items():
        assert (row - exact[p]).abs().max() < 1e-4, p


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_the_gated_unit(dtype):
    from damendaemon_b200 import kernels
    gate_up = rnd(13, 2 * 40, seed=12, scale=3.0).to(dtype)
    g = gate_up[:, :40].double().clamp(max=1.5)
    u = gate_up[:, 40:].double().clamp(-1.5, 1.5)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    got = kernels.gated_unit(gate_up.to(DEV), 1.5, 1.702).cpu().double()
    assert (got - want).abs().max() < (1e-5 if dtype == torch.float32 else 0.03)


@pytest.mark.parametrize("activation", ["relu2", None])
def test_relu_squared_in_the_products_epilogue(activation):
    from damendaemon_b200 import kernels
    a, w = rnd(70, 96, seed=13), rnd(200, 96, seed=14)
    want = a.double() @ w.double().T
    if activation:
        want = torch.relu(want) ** 2
    got = kernels.gemm_simt(a.to(DEV), w.to(DEV), activation=activation).cpu().double()
    assert (got - want).abs().max() < 1e-3
    ab, wb = a.to(torch.bfloat16), w.to(torch.bfloat16)
    want = ab.double() @ wb.double().T
    if activation:
        want = torch.relu(want) ** 2
    for rows in (70, 8):          # a tile of tokens, and the few-token product
        got = kernels.gemm_tcgen05(ab[:rows].to(DEV), wb.to(DEV), activation=activation, out_dtype=torch.float32).cpu().double()
        assert (got - want[:rows]).abs().max() < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,top,shared,tokens", [(6, 1, True, 1), (6, 1, True, 37), (4, 2, False, 200), (3, 3, True, 5), (16, 4, False, 70), (8, 2, False, 60)])
def test_experts_chosen_by_a_table(experts, top, shared, tokens, dtype):
    from damendaemon_b200.parts import GatedUnitSpec, Runtime, TableRoutedExpertsSpec
    from damendaemon_b200.parts.feed_forward import TableRoutedExperts
    from damendaemon_b200.engine.context import StepContext
    width, inner, vocab, limit = 64, 24, 50, 1.25
    names, w = {}, {}
    for e in list(range(experts)) + (["s"] if shared else []):
        p = "shared." if e == "s" else f"e{e}."
        size = 40 if e == "s" else inner
        w[p + "gate"], w[p + "up"] = rnd(size, width, seed=20 + len(w), scale=0.3), rnd(size, width, seed=21 + len(w), scale=0.3)
        w[p + "down"] = rnd(width, size, seed=22 + len(w), scale=0.3)
    g = torch.Generator().manual_seed(5)
    w["table"] = torch.rand((vocab, experts), generator=g).argsort(dim=1)[:, :top].contiguous()
    ids = torch.randint(0, vocab, (tokens,), generator=g)
    y, stream = rnd(tokens, width, seed=30), rnd(tokens, width, seed=31)
    rounded = {k: (t.to(dtype).double() if t.is_floating_point() else t) for k, t in w.items()}
    c = {"expert": {"limit": limit}, "shared": {"limit": 2.0} if shared else None}
    want = stream.double() + plain.table_routed_experts(y.to(dtype).double(), ids, rounded, c)
    unit = lambda p, lim, size: GatedUnitSpec(size, lim, p + "gate", p + "up", p + "down")
    spec = TableRoutedExpertsSpec("experts_by_table", width, vocab, top, "table", tuple(unit(f"e{e}.", limit, inner) for e in range(experts)),
                                  unit("shared.", 2.0, 40) if shared else None)
    runtime = Runtime(dtype=dtype, device=torch.device(DEV))
    weights = {k: (t.to(dtype) if t.is_floating_point() else t.to(torch.int32)).to(DEV) for k, t in w.items()}
    part = TableRoutedExperts(spec, weights, runtime)
    ctx = StepContext(n_tokens=tokens, n_entries=1, n_wanted=0, token_ids=ids.to(torch.int32).to(DEV), positions=None,
                      token_entry=None, want_rows=None, entry_slot=None, entry_start=None, entry_pos0=None, block_tables={},
                      runtime=runtime)
    got = part.forward(y.to(dtype).to(DEV), stream.clone().to(DEV), ctx).cpu().double()
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 0.05)

"""Zokanex on the CPU: configuration, the spec it becomes, tensor names, what a shared cache keeps, and the plain
implementation's own pieces (which the GPU tests then trust)."""
import copy

import pytest
import torch

import plain_zokanex as plain
from zokanex_tools import CONFIGS, TINY_P, TINY_Q, TINY_S, make_tensors, plain_tensors

from damendaemon_b200.config import ConfigError
from damendaemon_b200.parts import cache_needs, tensor_decls
from damendaemon_b200.registry import architecture_of


def spec_of(config):
    arch = architecture_of(config)
    return arch, arch.parse_config(config), arch.build_spec(arch.parse_config(config))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    config = CONFIGS[name]
    arch, typed, spec = spec_of(config)
    assert arch.name == "Zokanex"
    assert arch.parse_config(typed.to_dict()) == typed
    declared = set()
    for d in tensor_decls(spec):
        declared |= {n for n, _ in d.pieces} if d.pieces else {d.name}
    assert declared == set(arch.random_tensors(typed, 0))
    # every size of the random tensors is what the parts declare
    shapes = {}
    for d in tensor_decls(spec):
        shapes.update({n: tuple(s) for n, s in d.pieces} if d.pieces else {d.name: tuple(d.shape)})
    for n, t in arch.random_tensors(typed, 0).items():
        assert tuple(t.shape) == shapes[n], n


def test_a_layer_without_keys_reads_an_earlier_stop_and_the_cache_keeps_the_wider_window():
    _, typed, spec = spec_of(TINY_P)
    assert [e.cache_of for e in spec.run_order] == [None, 0, None, None, None]
    reader = spec.layers[1].mixer
    assert not reader.own_keys_values and reader.key_norm is None and reader.qkv_weight == ("l1.mix.q",)
    assert reader.window == 40 and spec.layers[0].mixer.window == 24 and spec.layers[0].mixer.keep_window == 40
    needs = cache_needs(spec)
    assert needs[1] == [] and needs[0][0].window == 40 and needs[4][0].window == 24
    assert needs[0][0].value_dim == 16 and needs[0][0].kv_heads == 2
    # retention asks for state rows, not pages
    assert type(needs[2][0]).__name__ == "RequestState" and needs[2][0].dtype == "float32" and needs[2][0].shape[0] == 2
    # a reader without a mask makes its source keep everything
    _, _, q = spec_of(TINY_Q)
    assert q.layers[2].mixer.keep_window == "all" and cache_needs(q)[2][0].window is None
    widened = copy.deepcopy(TINY_Q)
    widened["layers"][2]["mixer"]["mask"] = {"size": 5}
    assert cache_needs(spec_of(widened)[2])[2][0].window == 9


def test_the_constants_of_the_design_reach_the_specs():
    _, typed, spec = spec_of(TINY_S)
    a, f = spec.layers[0].mixer, spec.layers[0].feed_forward
    assert (a.n_heads, a.n_kv_heads, a.head_dim, a.value_dim, a.window) == (3, 1, 20, 12, 33)
    assert a.rotary.dims == 10 and a.rotary.base == 77.0 and not a.rotary.interleaved
    assert a.query_norm == "l0.mix.q.norm" and a.key_norm == "l0.mix.k.norm" and a.head_norm_eps == TINY_S["norm"]["eps"]
    assert (f.top, f.groups, f.keep_groups, f.weight_scale, len(f.experts)) == (2, 3, 1, 1.5, 6)
    assert f.experts[0].activation == "silu" and f.shared.inner == 12 and f.shared_gate == "l0.mlp.shared.sg"
    r = spec.layers[1].mixer
    assert r.decay == (0.98, 0.8) and r.key_scale == 40 ** -0.5 and r.rotary.dims == 20
    assert spec.layers[1].feed_forward.unit.activation == "gelu_tanh"
    assert all(layer.arrangement == "parallel" and len(layer.norms) == 1 for layer in spec.layers)
    assert spec.embedding.scale == 2.5 and spec.max_positions is None


@pytest.mark.parametrize("path,value,message", [
    (("layers", 1, "mixer", "kv_from"), 1, "kv_from"),
    (("layers", 1, "mixer", "kv_from"), 3, "kv_from"),
    (("layers", 1, "mixer", "dim"), 16, "other head sizes"),
    (("layers", 2, "mixer", "decay"), [0.5], "decay"),
    (("layers", 2, "mixer", "decay"), [0.5, 1.5], "decay"),
    (("layers", 0, "mixer", "rot", "dims"), 15, "rot.dims"),
    (("layers", 0, "mixer", "kv_heads"), 3, "cannot share"),
    (("layers", 1, "mlp", "router", "groups", "count"), 3, "groups"),
    (("layers", 1, "mlp", "router", "top"), 5, "can be chosen"),
    (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mlp", "kind"), "glu", "kind"),
    (("vocab",), 0, "vocab"),
])
def test_bad_fields_are_named(path, value, message):
    config = copy.deepcopy(TINY_P)
    at = config
    for key in path[:-1]:
        at = at[key]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        architecture_of(config).parse_config(config)


def test_a_reader_must_name_a_layer_with_keys_of_its_own():
    config = copy.deepcopy(TINY_P)
    config["layers"][4]["mixer"]["kv_from"] = 1          # layer 1 is a reader itself
    with pytest.raises(ConfigError, match="kv_from"):
        architecture_of(config).parse_config(config)
    config["layers"][4]["mixer"]["kv_from"] = 2          # a retention layer has no keys to lend
    with pytest.raises(ConfigError, match="kv_from"):
        architecture_of(config).parse_config(config)


# ---- the plain implementation's own pieces ----

def test_plain_retention_is_the_decayed_sum_it_claims():
    g = torch.Generator().manual_seed(1)
    T, H, dk, dv = 9, 2, 4, 3
    q, k, v = (torch.randn(T, H, d, generator=g, dtype=torch.float64) for d in (dk, dk, dv))
    decay = torch.tensor([0.9, 0.5], dtype=torch.float64)
    o, S = plain.retention_recurrence(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            want = sum(decay[h] ** (t - s) * (q[t, h] @ k[s, h]) * v[s, h] for s in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)
    # a portion continues from the state the portion before left
    o1, S1 = plain.retention_recurrence(q[:4], k[:4], v[:4], decay)
    o2, S2 = plain.retention_recurrence(q[4:], k[4:], v[4:], decay, S1)
    assert torch.allclose(torch.cat([o1, o2]), o, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)


def test_plain_window_and_rotation():
    see = plain.window_visible(6, 3)
    assert see[5].tolist() == [False, False, False, True, True, True] and see[1].tolist() == [True, True, False, False, False, False]
    assert plain.window_visible(4)[3].all()
    x = torch.arange(8, dtype=torch.float64).view(1, 1, 8) + 1
    out = plain.rotate_halves(x, torch.tensor([3]), 4, 100.0)
    # dimensions 0 and 2 form a pair, 1 and 3 another; 4..7 stay
    assert torch.equal(out[0, 0, 4:], x[0, 0, 4:])
    a = 3.0 * 100.0 ** (-2 * 1 / 4)
    assert out[0, 0, 1].item() == pytest.approx(2 * torch.cos(torch.tensor(a)).item() - 4 * torch.sin(torch.tensor(a)).item())
    assert out[0, 0, 3].item() == pytest.approx(4 * torch.cos(torch.tensor(a)).item() + 2 * torch.sin(torch.tensor(a)).item())
    # the score of a rotated pair depends on the distance only
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s1 = (plain.rotate_halves(q, torch.tensor([10]), 8, 50.0) * plain.rotate_halves(k, torch.tensor([7]), 8, 50.0)).sum()
    s2 = (plain.rotate_halves(q, torch.tensor([103]), 8, 50.0) * plain.rotate_halves(k, torch.tensor([100]), 8, 50.0)).sum()
    assert s1.item() == pytest.approx(s2.item(), abs=1e-9)


def test_plain_choice_of_experts():
    # two groups of three: the second group's two best sum higher although the single best score is in the first
    s = torch.tensor([[0.9, 0.1, 0.2, 0.6, 0.7, 0.05]], dtype=torch.float64)
    assert plain.choose_experts(s, 2, 2, 1).tolist() == [[4, 3]]
    assert plain.choose_experts(s, 2, 1, 1).tolist() == [[0, 4]]
    assert plain.choose_experts(s, 3, 2, 2).tolist() == [[0, 4, 3]]
    # groups of one: a group's worth is its only score
    assert plain.choose_experts(s, 2, 6, 2).tolist() == [[0, 4]]


def test_plain_forward_changes_when_a_mechanism_is_left_out():
    """Random weights must not hide a mechanism: leaving out the heads' norm weight, the shared expert's gate, the
    group limit or the retention's decay moves the logits far beyond any tolerance of the GPU tests."""
    config = TINY_P
    tensors = plain_tensors(make_tensors(config, 3))
    ids = list(range(3, 60))
    base = plain.forward(config, tensors, ids)
    for name, change in (("l0.mix.k.norm", lambda t: torch.ones_like(t)), ("l1.mlp.shared.sg", lambda t: t * 0),
                         ("l2.mix.g", lambda t: t * 0.5)):
        other = dict(tensors)
        other[name] = change(tensors[name])
        assert (plain.forward(config, other, ids) - base).abs().max() > 1e-2, name
    for path, value in ((("layers", 1, "mlp", "router", "groups"), {"count": 1, "keep": 1}), (("layers", 2, "mixer", "decay"), [0.8, 0.97]),
                        (("layers", 1, "mixer", "mask", "size"), 24), (("layers", 1, "mlp", "router", "scale"), 1.0)):
        other = copy.deepcopy(config)
        at = other
        for key in path[:-1]:
            at = at[key]
        at[path[-1]] = value
        assert (plain.forward(other, tensors, ids) - base).abs().max() > 1e-2, path

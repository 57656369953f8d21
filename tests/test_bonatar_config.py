"""Bonatar on the CPU: configuration, the spec it becomes, tensor names, the cache need of a chunked mask, and the
plain implementation's own pieces."""
import copy
import math

import pytest
import torch

import plain_bonatar as plain
from bonatar_tools import CONFIGS, TINY_P, TINY_Q, TINY_R, make_tensors, plain_tensors
from damendaemon_b200.cache import CacheManager
from damendaemon_b200.cache.manager import PagedKeyValues
from damendaemon_b200.config import ConfigError
from damendaemon_b200.parts import cache_needs, tensor_decls
from damendaemon_b200.registry import architecture_of


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_round_trip_and_tensor_names(name):
    config = CONFIGS[name]
    arch = architecture_of(config)
    typed = arch.parse_config(config)
    assert arch.parse_config(typed.to_dict()) == typed
    spec = arch.build_spec(typed)
    assert spec.max_positions is None and len(spec.run_order) == len(config["layers"])
    declared = set()
    for d in tensor_decls(spec):
        declared |= {n for n, _ in d.pieces} if d.pieces else {d.name}
    assert declared == set(arch.random_tensors(typed, 0))
    # an entry that runs another's tensors names that layer in the run order and has a cache of its own
    for stop, (entry, raw) in enumerate(zip(spec.run_order, config["layers"])):
        assert entry.cache_of is None
        if "weights_of" in raw:
            assert entry.layer == spec.run_order[raw["weights_of"]].layer
    assert all(needs for needs in cache_needs(spec))


def test_options_reach_the_parts():
    spec = architecture_of(TINY_P).build_spec(architecture_of(TINY_P).parse_config(TINY_P))
    m = spec.layers[0].mixer
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.value_dim, m.chunk) == (4, 2, 32, 16, 24)
    assert m.rotary.dims == 16 and m.rotary.interleaved and m.rotary.blend.factor == 4.0
    assert spec.layers[0].feed_forward.activation == "relu2"
    experts = spec.layers[1].feed_forward
    assert experts.top == 2 and len(experts.experts) == 4 and experts.shared.inner == 40 and experts.shared.limit == 2.5
    assert spec.embedding.scale == 8.0 and spec.head.norm.weight_offset == 1.0 and not spec.head.tied
    q = architecture_of(TINY_Q).build_spec(architecture_of(TINY_Q).parse_config(TINY_Q))
    assert q.layers[1].arrangement == "pre_norm_mixer" and len(q.layers) == 3 and q.run_order[3].layer == 1
    assert q.layers[0].feed_forward.shared is None and q.layers[0].mixer.rotary.blend is None
    r = architecture_of(TINY_R).build_spec(architecture_of(TINY_R).parse_config(TINY_R))
    assert r.layers[0].mixer.rotary is None and r.layers[0].mixer.chunk is None


@pytest.mark.parametrize("damage,word", [
    (lambda c: c["layers"][0].__setitem__("type", "recurrent"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "share"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 15), "even"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "other"), "kind"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "experts per token"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 2), "earlier layer"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 0), "another mixer or feed-forward"),
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].__setitem__("eps", 0), "eps"),
])
def test_a_bad_configuration_names_its_field(damage, word):
    config = copy.deepcopy(TINY_P)
    damage(config)
    with pytest.raises(ConfigError, match=word):
        architecture_of(config).parse_config(config)


def test_a_chunked_need_gives_pages_back_at_the_chunks_border():
    need = PagedKeyValues(2, 16, None, None, chunk=24)
    assert [need.first_needed(n) for n in (0, 23, 24, 25, 47, 48, 100)] == [0, 0, 24, 24, 24, 48, 96]
    assert need.span() == 23 and PagedKeyValues(2, 16, 10, None, 24).span() == 9
    assert PagedKeyValues(2, 16, None, 40).page_shape(8) == (2 * 8 * 56,)
    assert PagedKeyValues(2, 16, None, 16).page_shape(8) == (2, 2, 8, 16)
    assert need != PagedKeyValues(2, 16, None, None, chunk=25)          # another mask, another group of pages
    cache = CacheManager([[need], [need]], kv_tokens=64, page_size=8, max_requests=2, max_context=1000)
    cache.admit("a")
    held = []
    for length in range(1, 200):
        cache.extend([("a", length)])
        cache.advance("a", length)
        cache.check()
        table = cache.groups[0].tables["a"]
        first = (length - length % 24) // 8
        assert all(p == -1 for p in table[:first]) and all(p >= 0 for p in table[first:])
        held.append(cache.groups[0].pool.used_pages)
    assert max(held) <= 4           # a chunk of 24 touches at most four pages of 8
    cache.release("a")
    assert cache.used_tokens == 0


def test_plain_pieces():
    # no blending: plain powers of the base; blending: the ends of the ramp
    f, m = plain.rotary_frequencies(8, 100.0)
    assert torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 100 ** -0.5, 100 ** -0.75], dtype=torch.float64)) and m == 1.0
    f2, m2 = plain.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 0.5})
    assert f2[0] == f[0] and f2[-1] == pytest.approx(f[-1] / 4) and m2 == pytest.approx(0.1 * math.log(4.0) + 1)
    # rotation keeps lengths (times the factor) and leaves the rest of a head alone
    x = torch.randn(5, 2, 12, dtype=torch.float64)
    y = plain.rotate_pairs(x, torch.arange(5), f, 1.5)
    assert torch.allclose(y[..., :8].norm(dim=-1), 1.5 * x[..., :8].norm(dim=-1)) and torch.equal(y[..., 8:], x[..., 8:])
    assert torch.equal(plain.rotate_pairs(x, torch.zeros(5, dtype=torch.long), f, 1.0), x)
    see = plain.visible(7, 3)
    assert see[2].tolist() == [True, True, True, False, False, False, False]
    assert see[3].tolist() == [False, False, False, True, False, False, False]
    assert plain.visible(4)[3].all()


def test_plain_whole_model_is_causal_and_chunked():
    """Changing a token changes no earlier logits, and none after its chunk's end reaches... through attention only:
    with one-chunk layers a later chunk still sees it through nothing, so logits from the next chunk on are equal."""
    config = copy.deepcopy(TINY_Q)
    for layer in config["layers"]:
        if layer["mlp"] and layer["mlp"]["kind"] == "moe":
            layer["mlp"] = {"kind": "dense", "ff": 16}      # the table reads the token id itself
    tensors = plain_tensors(make_tensors(config, 3))
    ids = list(range(30))
    base = plain.forward(config, tensors, ids)
    other = list(ids)
    other[9] = 77
    moved = plain.forward(config, tensors, other)
    assert torch.equal(moved[:9], base[:9])
    assert not torch.allclose(moved[9:14], base[9:14])
    assert torch.allclose(moved[14:], base[14:])           # position 9 lies in chunk 7..13

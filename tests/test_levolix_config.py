"""Levolix without a device: the configuration reader and its refusals, the tensor list, what each
layer asks of the cache, and facts about the plain mechanisms that the device tests lean on."""
import copy

import numpy as np
import pytest

from levolix_helpers import CONFIGS, make_weights, SEEDS
from plain import levolix_plain as LP


def spec_of(cfg):
    from gguf2bin_b200.config import model_spec_from_dict
    return model_spec_from_dict(cfg)


def test_reader_takes_every_size_and_constant_from_the_configuration():
    spec = spec_of(CONFIGS["u"])
    assert (spec.architecture, spec.hidden_size, spec.vocab_size, len(spec.layers)) == ("Levolix", 64, 211, 3)
    assert spec.head.get("tied") is True and spec.final_norm.get("offset") == 1.0
    r = spec.layers[0]
    assert r.block.kind == "branch_norm" and r.norm.get("offset") == 1.0 and r.norm["eps"] == 1e-6
    m = r.mixer
    assert (m.kind, m["n_heads"], m["qk_dim"], m["v_dim"], m["decay"]) == ("retention", 3, 16, 24, (0.9, 0.97, 0.9995))
    assert (m["position"].kind, m["position"]["rotary_dim"], m["position"]["theta"]) == ("rope_neox", 8, 1e4)
    f = r.feed_forward
    assert (f.kind, f["n_experts"], f["n_identity"], f["top"], f["intermediate_size"]) == ("routed_experts", 5, 2, 3, 40)
    assert f.get("renormalise") is False and f.get("correction") is True
    left, right = (s for _, s in spec.layers[1].mixer["branches"])
    assert (left.kind, left["n_heads"], left["n_kv_heads"], left["head_dim"], left["v_dim"]) == ("gqa_attention", 4, 2, 16, 24)
    assert (left["chunk"], left["scale"], left["sink"], left["out_gate"], left["out_scale"]) == (16, 0.3, "zero", "sigmoid", 1.3)
    assert left["position"].kind == "rope_interleaved" and left["qk_norm_span"] == "projection" and left["bias"] is True
    assert (right.kind, right["n_heads"], right["n_qk_heads"], right["qk_dim"], right["v_dim"], right["conv_taps"],
            right["out_scale"]) == ("gated_delta", 4, 2, 16, 8, 3, 0.6)
    assert spec.layers[2].feed_forward is None


def test_tensor_list_matches_the_checkpoint_names():
    from gguf2bin_b200.engine.model import expected_tensors
    for name, cfg in CONFIGS.items():
        exp = expected_tensors(spec_of(cfg))
        have = make_weights(cfg, SEEDS[name])
        assert {k for k, e in exp.items() if not e.optional} == set(have) - {k for k, e in exp.items() if e.optional}
        for k, v in have.items():
            assert tuple(exp[k].shape) == v.shape, k


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="mamba"), "not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not a feed-forward"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18), "even and at most"),
    (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][1]["mixer"].pop("left_scale"), "left_scale"),
    (lambda c: c["norm"].pop("eps"), "norm.eps"),
    (lambda c: c.update(layers=[]), "non-empty"),
])
def test_refusals(change, message):
    from gguf2bin_b200.config import ConfigError
    cfg = copy.deepcopy(CONFIGS["u"])
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        spec_of(cfg)


def test_plain_mechanisms():
    rng = np.random.default_rng(0)
    # rotation: position 0 turns nothing; both layouts keep lengths; entries beyond ``dims`` pass
    x = rng.standard_normal((5, 2, 12))
    for inter in (False, True):
        y = LP.rotate(x, np.arange(5), 1e4, 8, inter)
        assert np.allclose(y[0], x[0]) and np.allclose(y[..., 8:], x[..., 8:])
        assert np.allclose((y * y).sum(-1), (x * x).sum(-1))
    assert not np.allclose(LP.rotate(x, np.arange(5), 1e4, 8, True), LP.rotate(x, np.arange(5), 1e4, 8, False))
    # the convolution: the last column weighs the current token, the tail carries over a cut
    w, xs = rng.standard_normal((3, 4)), rng.standard_normal((9, 3))
    whole, _ = LP.short_conv(xs, w, np.zeros((3, 3)))
    a, tail = LP.short_conv(xs[:4], w, np.zeros((3, 3)))
    b, _ = LP.short_conv(xs[4:], w, tail)
    assert np.allclose(np.concatenate([a, b]), whole) and np.allclose(whole[0], xs[0] * w[:, -1])
    # routing: identity experts return the input; the correction changes the choice, not the weights
    mlp = dict(expert=dict(ff=4), router=dict(experts=0, identity=3, top=3))
    W = {"r.router": rng.standard_normal((3, 6)), "r.correction": np.zeros(3)}
    h = rng.standard_normal((2, 6))
    assert np.allclose(LP.routed_ff(h, W, "r.", mlp), h)             # all three chosen: the weights sum to one
    mlp["router"]["top"] = 1
    z = h @ W["r.router"].T
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    W["r.correction"] = np.array([0.0, 0.0, 5.0])
    assert np.allclose(LP.routed_ff(h, W, "r.", mlp), h * s[:, 2:3])


def test_cache_needs_of_the_layers():
    torch = pytest.importorskip("torch")
    from gguf2bin_b200.cache.storage import KVNeed, StateNeed
    from gguf2bin_b200.parts import mixer_class
    spec = spec_of(CONFIGS["u"])
    m0 = spec.layers[0].mixer
    part = mixer_class(m0)(m0, 64, torch.float32, "cpu")
    assert part.cache_need() == StateNeed((3, 24, 16), torch.float32)
    m1 = spec.layers[1].mixer
    need = mixer_class(m1)(m1, 64, torch.bfloat16, "cpu").cache_need()
    assert need == {"left": KVNeed(2, 24, 0), "right.state": StateNeed((4, 8, 16), torch.float32),
                    "right.conv": StateNeed((3, 2 * 2 * 16 + 4 * 8), torch.bfloat16, by_position=True)}

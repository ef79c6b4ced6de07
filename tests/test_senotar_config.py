"""Senotar without a device: the configuration reader and what it refuses, the tensor list
against the weights the tests make, the cache's named needs, and a few facts about the plain
implementation's mechanisms that do not need a second implementation to state."""
import copy

import numpy as np
import pytest
import torch

from senotar_helpers import CONFIGS, make_weights
from plain import senotar_plain as SP


def spec_of(cfg):
    from gguf2bin_b200.config import model_spec_from_dict
    return model_spec_from_dict(cfg)


def test_every_size_and_constant_comes_from_the_configuration():
    spec = spec_of(CONFIGS["q"])
    assert spec.architecture == "Senotar" and spec.hidden_size == 96 and spec.vocab_size == 257
    assert [e.cache_of for e in spec.schedule] == [None, 0, None, 0]
    m = spec.layers[1].mixer
    assert (m["n_heads"], m["qk_dim"], m["v_dim"], m["kv_rank"], m["shared_kv"]) == (3, 8, 40, 64, True)
    assert spec.layers[0].mixer["scale"] == 0.3 and spec.layers[0].block["conv_taps"] == 2
    assert spec.embedding["buckets"] == 97 and spec.embedding["eps"] == 1e-5
    assert spec_of(CONFIGS["p"]).layers[1].feed_forward is None


def test_the_tensor_list_is_the_checkpoints():
    from gguf2bin_b200.engine import expected_tensors
    for name, cfg in CONFIGS.items():
        want = {k: tuple(e.shape) for k, e in expected_tensors(spec_of(cfg)).items() if not e.optional}
        have = {k: tuple(v.shape) for k, v in make_weights(cfg, 0).items()}
        assert want == have, name


@pytest.mark.parametrize("change,words", [
    (lambda c: c["layers"][0].update(type="window_attention"), "is not a mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "is not a feed-forward"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "no\nlatents of its own".replace("\n", " ")),
    (lambda c: c["layers"][1]["mixer"].update(kv_rank=32), "differs from layer 0"),
    (lambda c: c["canon"].pop("taps"), "canon.taps"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "at least 1"),
    (lambda c: c.pop("width"), "width"),
])
def test_what_the_reader_refuses(change, words):
    from gguf2bin_b200.config import ConfigError
    cfg = copy.deepcopy(CONFIGS["q"])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        spec_of(cfg)
    assert words in str(e.value)


def test_named_needs_and_borrowed_storage():
    """A position may need pages AND a ring; a borrower keeps its own ring and reads the owner's pages."""
    from gguf2bin_b200.cache import Cache, KVNeed, StateNeed
    ring = StateNeed((3, 4), torch.float32, by_position=True)
    needs = [{"mixer": KVNeed(1, 8, 0, planes=1), "conv": ring}, {"conv": ring},
             StateNeed((2,), torch.int32, by_position=True)]
    cache = Cache(needs, max_tokens=256, dtype=torch.float32, device="cpu", max_seqs=5)
    pages = cache.view(0)["mixer"]
    assert pages.planes == 1 and tuple(pages.pages.shape) == (4 + 1, 1, 1, 64, 8)
    assert tuple(cache.view(0)["conv"].states.shape) == (5 + 1, 3, 4)
    assert cache.view(1)["conv"].states.data_ptr() != cache.view(0)["conv"].states.data_ptr()
    lent = cache.view_for(1, 0)
    assert lent["mixer"].pages.data_ptr() == pages.pages.data_ptr()
    assert lent["conv"].states.data_ptr() == cache.view(1)["conv"].states.data_ptr()
    assert cache.view(2).states.dtype == torch.int32
    # a slot that is opened again starts with cleared rings
    seq = cache.open_sequence()
    slot = seq.slot
    cache.view(0)["conv"].states[slot] = 7.0
    cache.close_sequence(seq)
    again = cache.open_sequence()
    assert again.slot == slot and float(cache.view(0)["conv"].states[again.slot].abs().sum()) == 0.0
    # pages with two panels are another group than pages with one
    assert KVNeed(1, 8).group_key != KVNeed(1, 8, planes=1).group_key


def test_plain_mechanisms():
    rng = np.random.default_rng(0)
    # a sink far below every score leaves the ordinary softmax; a sink far above takes everything
    q, k, v = rng.standard_normal((5, 8)), rng.standard_normal((5, 8)), rng.standard_normal((5, 3))
    plain = SP.sink_softmax_attention(q, k, v, 0.5, -1e9)
    s = np.where(np.tril(np.ones((5, 5), bool)), (q @ k.T) * 0.5, -np.inf)
    p = np.exp(s - s.max(1, keepdims=True))
    assert np.allclose(plain, (p / p.sum(1, keepdims=True)) @ v)
    assert np.abs(SP.sink_softmax_attention(q, k, v, 0.5, 60.0)).max() < 1e-15
    # with equal scores the sink at the same height counts as one more key
    one = SP.sink_softmax_attention(np.zeros((3, 4)), k[:3, :4], np.ones((3, 2)), 1.0, 0.0)
    assert np.allclose(one[:, 0], [1 / 2, 2 / 3, 3 / 4])
    # the convolution of an impulse is the filter, newest tap last
    h = np.zeros((6, 2))
    h[1] = 1.0
    w = np.array([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    assert np.allclose(SP.causal_conv(h, w)[:, 0], [0, 3, 2, 1, 0, 0])
    assert np.allclose(SP.causal_conv(h, w)[:, 1], [0, 6, 5, 4, 0, 0])
    # the activation is continuous at zero with slope one half on both sides
    e = 1e-6
    assert abs(SP.xielu(np.array(e), 0.3, -0.2) - SP.xielu(np.array(-e), 0.3, -0.2) - e) < 1e-9
    # rows of the pair table: the first token takes the extra row, the others a hash of two ids
    assert SP.bigram_rows([5, 9, 9], 11, 3, 2) == [11, (5 * 3 + 9 * 2) % 11, (9 * 3 + 9 * 2) % 11]


def test_the_plain_model_does_not_care_how_long_the_sequence_is():
    """Causality: the logits of a prefix are those of the longer sequence's first rows."""
    cfg, W = CONFIGS["p"], make_weights(CONFIGS["p"], 3)
    toks = np.random.default_rng(1).integers(0, cfg["vocab"], 12).tolist()
    full, part = SP.forward(cfg, W, toks), SP.forward(cfg, W, toks[:7])
    assert np.abs(full[:7] - part).max() < 1e-10
